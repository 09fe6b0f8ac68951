"""Seeded random shapes on the two tensor-core families, every weight type: ragged N (any value, not a multiple of the
16-row / 128-row tiles), K at every multiple the type's row alignment allows (so the last K chunk of a stage is partial
and, for the types whose blocks are not 16-byte multiples, every phase of a block inside its aligned window occurs),
every M of the family.  Against the CPU oracle, through the C ABI."""
import numpy as np
import pytest
import torch

import oracle
from dinoml_v2_b200 import kernels, synthetic as S

pytestmark = pytest.mark.gpu
TDT = {"float16": torch.float16, "bfloat16": torch.bfloat16}
K_STEP = {"Q4_K": 256, "Q5_K": 256, "Q8_0": 256, "Q4_0": 256, "NVFP4": 256, "MXFP4": 512, "Q2_K": 1024, "Q6_K": 2048, "Q3_K": 2048}


def _cases(qtype, family, count, seed):
    rng = np.random.Generator(np.random.PCG64(seed))
    step = K_STEP[qtype]
    for _ in range(count):
        m = int(rng.integers(1, 9)) if family == "stream" else int(rng.choice([9, 16, 17, 40, 64, 65, 128, 129, 200, 257, 300]))
        n = int(rng.integers(1, 700))
        k = step * int(rng.integers(1, max(2, 6144 // step) + 1))
        yield m, n, k


@pytest.mark.parametrize("dtype", ["bfloat16", "float16"])
@pytest.mark.parametrize("qtype", sorted(K_STEP))
def test_random_shapes_on_the_persistent_gemv(qtype, dtype):
    if qtype == "Q8_0":
        pytest.skip("Q8_0 decode runs on the tile GEMV")
    dev = torch.device("cuda:0")
    bound = 4e-3 if dtype == "bfloat16" else 6e-4        # output rounding of bf16 (2^-9) / fp16 (2^-11)
    for i, (m, n, k) in enumerate(_cases(qtype, "stream", 8, 5100 + len(qtype))):
        blocks = S.random_blocks(qtype, n, k, seed=5200 + i)
        x = torch.from_numpy(S.random_activations(m, k, 5300 + i, "float32")).to(dev).to(TDT[dtype])
        ref = oracle.gemm_quant(x.float().cpu().numpy(), blocks, qtype, n, k)
        variant = "stream" if i % 2 == 0 else f"stream:{1 + i % 4}"
        y = kernels.gemm_rcr(x, torch.from_numpy(blocks).to(dev), qtype, variant=variant)
        assert kernels.device_status() == 0, (qtype, variant, m, n, k)
        got = y.float().cpu().numpy()
        assert np.isfinite(got).all()
        _, rel, norm = oracle.max_errors(ref, got)
        assert norm <= bound and rel <= (2e-2 if dtype == "bfloat16" else 1e-3), (qtype, dtype, variant, m, n, k, rel, norm)


@pytest.mark.parametrize("dtype", ["bfloat16", "float16"])
@pytest.mark.parametrize("qtype", sorted(K_STEP))
def test_random_shapes_on_the_tcgen05_gemm(qtype, dtype):
    dev = torch.device("cuda:0")
    tol = 2e-2 if dtype == "bfloat16" else 1e-3
    for i, (m, n, k) in enumerate(_cases(qtype, "umma", 6, 5400 + len(qtype))):
        blocks = S.random_blocks(qtype, n, k, seed=5500 + i)
        x = torch.from_numpy(S.random_activations(m, k, 5600 + i, "float32")).to(dev).to(TDT[dtype])
        xf = x.float().cpu().numpy()
        ref = oracle.gemm_quant(xf, blocks, qtype, n, k)
        y = kernels.gemm_rcr(x, torch.from_numpy(blocks).to(dev), qtype, variant="umma")
        assert kernels.device_status() == 0, (qtype, m, n, k)
        got = y.float().cpu().numpy()
        assert np.isfinite(got).all()
        _, _, norm = oracle.max_errors(ref, got)
        assert norm <= tol, (qtype, dtype, m, n, k, norm)
        assert oracle.within_operand_noise(ref, got, oracle.dot_noise(xf, blocks, qtype, k), dtype, tol), (qtype, dtype, m, n, k)
