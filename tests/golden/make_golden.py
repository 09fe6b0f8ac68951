"""Generates the committed golden fixtures.  Run in a container that has the reference tree
(path argument, else $DINOML_REFERENCE_DIR, else the build container's default location) and the third-party `gguf` package; the fixtures then travel with
the repository and the tests never need either again.

  python tests/golden/make_golden.py [/path/to/reference]

Fixtures written next to this script:

* gguf_dequant_kat.npz - per qtype a handful of hand-built edge-case blocks (zero / subnormal /
  maximal / negative fp16 scales, all-zero and all-max quants, extreme sub-block scales) plus
  seeded random blocks, with the expected dequantized values as raw fp32 / fp16 / bf16 bit
  patterns.  Expected values come from the C oracle and are asserted bit-identical to the numpy
  twin AND to `gguf.quants.dequantize` (independent implementation) before they are saved.
* gemm_rcr_reference_cpu.npz - small quantized linears pushed through the REFERENCE ITSELF:
  `dml.compile(spec, dml.Target("cpu"))` of a one-node `dml.ops.gemm_rcr` graph whose constant is
  the host-dequantized weight (what GGUFConstant.materialize produces on the CPU target,
  src/dinoml/constant_sources.py:58-79), run with `Session.run_numpy`.  Inputs, GGUF blocks and
  the reference's outputs are stored.
"""
from __future__ import annotations

import os
import sys
import tempfile
from pathlib import Path

import numpy as np

HERE = Path(__file__).resolve().parent
ROOT = HERE.parent.parent
sys.path.insert(0, str(ROOT))

import oracle  # noqa: E402
from dinoml_v2_b200 import synthetic as S  # noqa: E402
from oracle import build_ref  # noqa: E402

F16_EDGE = np.array([0x0000, 0x0001, 0x03FF, 0x0400, 0x7BFF, 0x8001, 0xBC00, 0x3C00], dtype=np.uint16).view(np.float16)


def edge_blocks(qtype: str) -> np.ndarray:
    """One row of 8 edge-case blocks + a second row of 8 random ones."""
    rng = np.random.Generator(np.random.PCG64(99))
    n = len(F16_EDGE)
    if qtype == "Q8_0":
        qs = rng.integers(-127, 128, size=(n, 32), dtype=np.int8)
        qs[0] = 0
        qs[1] = 127
        qs[2] = -128
        return S.pack_q8_0(F16_EDGE, qs).reshape(1, -1)
    if qtype == "Q4_K":
        sc = rng.integers(0, 64, size=(n, 8), dtype=np.uint8)
        mn = rng.integers(0, 64, size=(n, 8), dtype=np.uint8)
        q = rng.integers(0, 16, size=(n, 256), dtype=np.uint8)
        sc[0], mn[0], q[0] = 0, 0, 0
        sc[1], mn[1], q[1] = 63, 63, 15
        sc[2], mn[2] = 63, 0
        sc[3], mn[3] = 0, 63
        return S.pack_q4_k(F16_EDGE, F16_EDGE[::-1].copy(), sc, mn, q).reshape(1, -1)
    if qtype == "Q6_K":
        scales = rng.integers(-128, 128, size=(n, 16), dtype=np.int8)
        q = rng.integers(0, 64, size=(n, 256), dtype=np.uint8)
        scales[0], q[0] = 0, 0
        scales[1], q[1] = 127, 63
        scales[2], q[2] = -128, 0
        scales[3] = -128
        return S.pack_q6_k(F16_EDGE, scales, q).reshape(1, -1)
    # the further types: random bytes everywhere, then the edge scales and extreme quant fields in the first blocks
    q = S.qtype_of(qtype)
    blocks = rng.integers(0, 256, size=(n, q.block_bytes), dtype=np.uint8)
    if qtype == "MXFP4":
        blocks[:, 0] = np.array([0, 1, 2, 117, 127, 200, 254, 255], dtype=np.uint8)      # e8m0 exponents incl. the two sub-2 cases
        blocks[0, 1:] = 0x00
        blocks[1, 1:] = 0xFF
        blocks[2, 1:] = 0x7F
    elif qtype == "NVFP4":
        blocks[:, 0:4] = np.array([[0x00, 0x7F, 0x01, 0x07], [0x08, 0x38, 0x7E, 0xFF], [0x80, 0x47, 0x20, 0x30]] + [[32, 40, 48, 56]] * 5,
                                  dtype=np.uint8)
        blocks[0, 4:] = 0x00
        blocks[1, 4:] = 0xFF
    else:
        for off in S._HALF_FIELDS[qtype]:
            blocks[:, off:off + 2] = F16_EDGE[:, None].view(np.uint8)
        lo = {"Q4_0": 2, "Q5_K": 4, "Q2_K": 0, "Q3_K": 0}[qtype]
        hi = {"Q4_0": 18, "Q5_K": 176, "Q2_K": 80, "Q3_K": 108}[qtype]
        blocks[0, lo:hi] = 0x00
        blocks[1, lo:hi] = 0xFF
    return blocks.reshape(1, -1)


def reference_host_dequantize(blocks: np.ndarray, qtype: str, k: int):
    """The reference's own `<qtype>_value_host` functions (oracle/_ref/libref_gguf_host.so, built by oracle/build_ref.py), or None."""
    import ctypes
    path = ROOT / "oracle" / "_ref" / "libref_gguf_host.so"
    if not path.exists():
        return None
    lib = ctypes.CDLL(str(path))
    out = np.empty((blocks.shape[0], k), dtype=np.float32)
    rc = lib.ref_gguf_dequantize_rows(blocks.ctypes.data_as(ctypes.c_void_p), oracle.QTYPE_VALUE[qtype], ctypes.c_int64(blocks.shape[0]),
                                      ctypes.c_int64(k), out.ctypes.data_as(ctypes.c_void_p))
    assert rc == 0, rc
    return out


def make_dequant_kat() -> None:
    import gguf
    from gguf import GGMLQuantizationType as T

    out = {}
    for i, qtype in enumerate(("Q8_0", "Q4_K", "Q6_K", "Q4_0", "Q5_K", "Q2_K", "Q3_K", "MXFP4", "NVFP4")):
        bs = oracle.BLOCK[oracle.QTYPE_VALUE[qtype]][0]
        k = 8 * bs
        blocks = np.concatenate([edge_blocks(qtype), S.random_blocks(qtype, 3, k, seed=4100 + i)], axis=0)
        w = oracle.dequantize(blocks, qtype, k, "float32")
        w_gg = gguf.quants.dequantize(blocks, getattr(T, qtype)).astype(np.float32)
        if qtype in ("Q8_0", "Q4_K", "Q6_K"):
            assert np.array_equal(w.view(np.uint32), oracle.dequantize_numpy(blocks, qtype, k).view(np.uint32)), qtype
        assert np.array_equal(w.view(np.uint32), w_gg.view(np.uint32)), qtype
        ref = reference_host_dequantize(blocks, qtype, k)
        assert ref is None or np.array_equal(w.view(np.uint32), ref.view(np.uint32)), qtype
        out[f"{qtype}_blocks"] = blocks
        out[f"{qtype}_n_per_row"] = np.int64(k)
        out[f"{qtype}_f32_bits"] = w.view(np.uint32)
        out[f"{qtype}_f16_bits"] = oracle.dequantize(blocks, qtype, k, "float16").view(np.uint16)
        out[f"{qtype}_bf16_bits"] = oracle.dequantize(blocks, qtype, k, "bfloat16")
        # fp16 expectation cross-checked with numpy's own RNE cast
        assert np.array_equal(out[f"{qtype}_f16_bits"], w.astype(np.float16).view(np.uint16)), qtype
    np.savez_compressed(HERE / "gguf_dequant_kat.npz", **out)
    print("wrote gguf_dequant_kat.npz", {k: v.shape for k, v in out.items() if hasattr(v, "shape") and v.ndim})


def run_reference_cpu(reference: Path, x: np.ndarray, w_dense: np.ndarray, dtype: str, workdir: Path) -> np.ndarray:
    """x / w_dense are float32 arrays; the reference stores them in `dtype`."""
    sys.path.insert(0, str(reference / "src"))
    os.environ["DINOML_CACHE_DIR"] = str(workdir / "cache")
    import dinoml as dml
    from dinoml import runtime

    n, k = w_dense.shape

    class Lin(dml.Module):
        def __init__(self):
            super().__init__()
            self.weight = dml.Parameter([n, k], dtype=dtype)

        def forward(self, x):
            return dml.ops.gemm_rcr(x, self.weight)

    spec = dml.trace(Lin(), inputs={"x": dml.TensorSpec(list(x.shape), dtype)}, constants={"weight": w_dense})
    art = workdir / f"art_{dtype}_{x.shape[0]}_{n}_{k}"
    dml.compile(spec, dml.Target("cpu"), art)
    mod = runtime.load(art)
    sess = mod.create_session()
    out = sess.run_numpy({"x": x})
    return np.asarray(list(out.values())[0])


def make_gemm_golden(reference: Path) -> None:
    cases = [  # (qtype, dtype, m, n, k)
        ("Q8_0", "float32", 1, 48, 256),
        ("Q8_0", "float32", 3, 40, 512),
        ("Q4_K", "bfloat16", 1, 48, 512),
        ("Q4_K", "bfloat16", 5, 40, 1024),
        ("Q6_K", "bfloat16", 4, 24, 768),
        ("Q6_K", "float32", 2, 24, 512),
        ("Q4_K", "float16", 2, 32, 512),
        ("Q4_K", "bfloat16", 4, 512, 4096),
        ("Q6_K", "bfloat16", 64, 256, 2048),
    ]
    out = {"cases": np.array(["|".join(map(str, c)) for c in cases])}
    with tempfile.TemporaryDirectory() as tmp:
        for i, (qtype, dtype, m, n, k) in enumerate(cases):
            blocks = S.random_blocks(qtype, n, k, seed=5200 + i)
            x = S.random_activations(m, k, 5300 + i, "float32")
            w = oracle.dequantize(blocks, qtype, k, "float32")
            y = run_reference_cpu(reference, x, w, dtype, Path(tmp))
            # the reference returns float32 views of its storage dtype for 16-bit types
            key = f"case{i}"
            out[f"{key}_blocks"] = blocks
            out[f"{key}_x_f32"] = x
            out[f"{key}_y"] = np.asarray(y)
            # sanity: agree with float64 math on the dtype-rounded operands
            if dtype == "bfloat16":
                xr = S.bf16_bits_to_float32(S.float32_to_bf16_bits(x))
                wr = S.bf16_bits_to_float32(S.float32_to_bf16_bits(w))
                tol = 2e-2
            elif dtype == "float16":
                xr, wr, tol = x.astype(np.float16).astype(np.float32), w.astype(np.float16).astype(np.float32), 3e-3
            else:
                xr, wr, tol = x, w, 1e-5
            ref64 = xr.astype(np.float64) @ wr.astype(np.float64).T
            yf = np.asarray(y, dtype=np.float64)
            err = np.abs(yf - ref64).max() / np.abs(ref64).max()
            print(key, qtype, dtype, (m, n, k), "y dtype", np.asarray(y).dtype, "norm err vs f64", err)
            assert err < tol, (key, err)
    np.savez_compressed(HERE / "gemm_rcr_reference_cpu.npz", **out)
    print("wrote gemm_rcr_reference_cpu.npz")


if __name__ == "__main__":
    ref = Path(sys.argv[1]) if len(sys.argv) > 1 else Path(os.environ.get("DINOML_REFERENCE_DIR", os.sep + os.path.join("root", "reference")))
    build_ref.build(ref)                      # the reference-authored decode functions the vectors are checked against
    make_dequant_kat()
    make_gemm_golden(ref)
