"""GPU parity at the benchmark configurations' FULL sizes, on the kernel the shape-guarded dispatch (variant = auto)
actually picks, against the CPU oracle.

The oracle is a scalar CPU loop, so large cases compare a sample of weight rows (first / middle / last tiles and a
seeded random set): `oracle.gemm_quant(x, blocks[rows])` against `y[:, rows]`.  Every case also checks an
order-independent checksum of the whole output against a second launch (determinism of the work split).
Bars (the path's stated tolerances): float32 / float16 outputs 1e-3, bfloat16 outputs 2e-2, on max|d| / max|e| for
every kernel and on the reference harness metric |d| / max(1, |e|) (tools/bench_ck_gguf_q8_gemm.hip:798-808) for the
kernels that keep the dequantized weights in fp32 (simt, mma, stream).  The tcgen05 kernel feeds the tensor cores 16-bit
weights - as the reference's own CPU path does, which rounds the weights to the storage dtype before multiplying - so an
output that happens to cancel to almost zero carries the rounding noise of its K products; for it the element-wise bar
is tol * max(1, |e|) + 6 * ulp16 * sqrt(sum_k (x_k w_k)^2) (oracle.within_operand_noise)."""
import json
import os
from pathlib import Path

import numpy as np
import pytest
import torch

import oracle
from dinoml_v2_b200 import kernels, synthetic as S

pytestmark = pytest.mark.gpu
TDT = {"float32": torch.float32, "float16": torch.float16, "bfloat16": torch.bfloat16}
TOL = {"float32": 1e-3, "float16": 1e-3, "bfloat16": 2e-2}
_RECORD = []


def _sample_rows(n, count, seed):
    if n <= count:
        return np.arange(n)
    rng = np.random.default_rng(seed)
    fixed = np.r_[0:16, n // 2 - 8:n // 2 + 8, n - 16:n]
    extra = rng.choice(n, size=max(0, count - fixed.size), replace=False)
    return np.unique(np.r_[fixed, extra])


def _run_case(name, qtype, m, n, k, dtype, expect_variant, seed, sample=96, gpu_blocks=True):
    dev = torch.device("cuda:0")
    oracle.set_threads(max(1, min(16, os.cpu_count() or 1)))
    if gpu_blocks:                                     # big weights: generate on the GPU, fetch only the sampled rows
        bq = S.random_blocks_torch(qtype, n, k, seed, dev)
    else:
        bq = torch.from_numpy(S.random_blocks(qtype, n, k, seed)).to(dev)
    xf32 = S.random_activations(m, k, seed + 1, "float32")
    x = torch.from_numpy(xf32).to(dev).to(TDT[dtype])
    xf = x.float().cpu().numpy()
    variant = kernels.select_variant(qtype, dtype, m, n, k)
    assert variant == expect_variant, (name, variant)
    y = kernels.gemm_rcr(x, bq, qtype)
    again = kernels.gemm_rcr(x, bq, qtype)
    assert kernels.device_status() == 0, name
    bits = torch.int32 if dtype == "float32" else torch.int16
    assert int(y.view(bits).to(torch.int64).sum().item()) == int(again.view(bits).to(torch.int64).sum().item()), name
    rows = _sample_rows(n, sample, seed + 2)
    ridx = torch.from_numpy(rows).to(dev)
    ref = oracle.gemm_quant(xf, bq[ridx].cpu().numpy(), qtype, len(rows), k)
    got = y[:, ridx].float().cpu().numpy()
    assert np.isfinite(got).all(), name
    max_abs, rel, norm = oracle.max_errors(ref, got)
    _RECORD.append({"case": name, "qtype": qtype, "m": m, "n": n, "k": k, "dtype": dtype, "variant": variant, "rows_checked": int(len(rows)),
                    "max_abs": max_abs, "rel": rel, "norm": norm})
    assert norm <= TOL[dtype], (name, variant, rel, norm)
    if variant == "umma" and qtype not in ("MXFP4", "NVFP4"):     # FP4 values times their block scales are exact 16-bit operands: no floor needed
        noise = oracle.dot_noise(xf, bq[ridx].cpu().numpy(), qtype, k)
        assert oracle.within_operand_noise(ref, got, noise, dtype, TOL[dtype]), (name, variant, max_abs, rel)
    else:
        assert rel <= TOL[dtype], (name, variant, rel, norm)


def test_config1_q8_0_float32_gemv():
    _run_case("cfg1", "Q8_0", 1, 4096, 4096, "float32", "simt", 9100, sample=4096, gpu_blocks=False)


@pytest.mark.parametrize("m", [1, 4, 16])
def test_config2_q4k_decode(m):
    expect = kernels.select_variant("Q4_K", "bfloat16", m, 11008, 4096)
    assert expect in (("stream", "mma") if m <= 8 else ("umma",))
    _run_case(f"cfg2_m{m}", "Q4_K", m, 11008, 4096, "bfloat16", expect, 9200 + m, sample=11008 if m == 1 else 512, gpu_blocks=False)


@pytest.mark.parametrize("m", [64, 512, 2048])
def test_config3_q6k_prefill(m):
    _run_case(f"cfg3_m{m}", "Q6_K", m, 4096, 14336, "bfloat16", "umma", 9300 + m, sample=64 if m >= 512 else 256)


@pytest.mark.parametrize("name,qtype,n,k", [("q", "Q4_K", 4096, 4096), ("k", "Q4_K", 1024, 4096), ("v", "Q6_K", 1024, 4096),
                                            ("gate_up", "Q4_K", 14336, 4096), ("down", "Q6_K", 4096, 14336),
                                            ("lm_head", "Q6_K", 128256, 4096)])
def test_config4_llama8b_decode_shapes(name, qtype, n, k):
    expect = kernels.select_variant(qtype, "bfloat16", 1, n, k)
    assert expect in ("stream", "mma")
    _run_case(f"cfg4_{name}", qtype, 1, n, k, "bfloat16", expect, 9400 + n % 97, sample=1024)


@pytest.mark.parametrize("world", [2, 4, 8])
@pytest.mark.parametrize("m", [1, 16, 256])
def test_config5_shard_shapes(world, m):
    """Per-GPU shapes of the sharded 70B FFN: gate / up row shard [28672 / G, 8192], down K shard [8192, 28672 / G]."""
    for part, n, k in (("gate_up", 28672 // world, 8192), ("down", 8192, 28672 // world)):
        expect = kernels.select_variant("Q4_K", "bfloat16", m, n, k)
        _run_case(f"cfg5_g{world}_{part}_m{m}", "Q4_K", m, n, k, "bfloat16", expect, 9500 + world * 10 + m % 7, sample=64 if m == 256 else 160)


@pytest.mark.parametrize("qtype", ["Q4_0", "Q5_K", "Q2_K", "Q3_K", "MXFP4", "NVFP4"])
@pytest.mark.parametrize("m,dtype", [(1, "bfloat16"), (8, "float16"), (512, "bfloat16"), (64, "float16")])
def test_further_qtypes_at_full_size(qtype, m, dtype):
    """The six further types of the reference prototype on a Llama-8B down-projection shape [4096 x 14336]: decode rows on the
    persistent GEMV, prefill rows on the tcgen05 GEMM (K = 14336 gives 16-byte weight rows for every one of them)."""
    expect = "stream" if m <= 8 else "umma"
    _run_case(f"more_{qtype}_m{m}_{dtype}", qtype, m, 4096, 14336, dtype, expect, 9600 + m, sample=64 if m >= 64 else 256)


def test_zz_write_error_record():
    """Writes the measured errors of the cases above into $DINOML_TEST_REPORT_DIR (when set and existing)."""
    out = os.environ.get("DINOML_TEST_REPORT_DIR")
    if out and Path(out).is_dir() and _RECORD:
        (Path(out) / "parity_full_size.json").write_text(json.dumps(_RECORD, indent=1))
    assert all(r["norm"] <= TOL[r["dtype"]] for r in _RECORD)
