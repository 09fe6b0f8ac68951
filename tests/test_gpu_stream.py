"""GPU parity tests of the persistent bulk-copy GEMV ("stream" variant), through the C ABI, against the CPU oracle.

Covers every tuning configuration, both 16-bit dtypes, every M bucket, ragged N (last tile partly outside the weight),
fewer tiles than SMs and many more, K of one chunk (groups that get no stage in some tiles), K with a partial last
chunk, bias, the gated epilogue and the scatter epilogue."""
import ctypes

import numpy as np
import pytest
import torch

import oracle
from dinoml_v2_b200 import _native, kernels, synthetic as S

pytestmark = pytest.mark.gpu
TDT = {"float16": torch.float16, "bfloat16": torch.bfloat16}


def _x(m, k, seed, dtype, dev):
    xt = torch.from_numpy(S.random_activations(m, k, seed, "float32")).to(dev).to(TDT[dtype])
    return xt, xt.float().cpu().numpy()


def _configs():
    return ["stream"] + [f"stream:{c}" for c in range(1, kernels.variant_configs("stream") + 1)]


@pytest.mark.parametrize("dtype", ["bfloat16", "float16"])
@pytest.mark.parametrize("qtype", ["Q4_K", "Q6_K", "Q5_K", "Q4_0", "MXFP4", "NVFP4", "Q2_K", "Q3_K"])
def test_stream_gemv_against_oracle(dtype, qtype):
    dev = torch.device("cuda:0")
    shapes = [(1, 16, 256), (1, 1000, 1024), (2, 50, 512), (3, 129, 4096), (4, 128, 4096), (5, 4000, 2048), (7, 33, 768), (8, 64, 2048),
              (1, 2400, 4096), (2, 5000, 11008), (8, 2368, 6144), (1, 7, 512)]
    if qtype == "Q6_K":                                   # 16-byte row pieces need K % 2048 == 0; other K stay with the tile kernel
        assert not kernels.variant_supports("stream", "Q6_K", dtype, 1, 64, 1024)
        shapes = [(m, n, -(-k // 2048) * 2048) for (m, n, k) in shapes] + [(1, 4096, 14336), (4, 300, 14336)]
    if qtype in ("MXFP4", "Q2_K", "Q3_K"):                # 136 / 84 / 110 bytes per 256 weights: 16-byte rows need K % 512 / 1024 / 2048 == 0
        step = {"MXFP4": 512, "Q2_K": 1024, "Q3_K": 2048}[qtype]
        assert not kernels.variant_supports("stream", qtype, dtype, 1, 64, 768)
        shapes = [(m, n, -(-k // step) * step) for (m, n, k) in shapes]
    for (m, n, k) in shapes:
        blocks = S.random_blocks(qtype, n, k, seed=2500 + m + n)
        bq = torch.from_numpy(blocks).to(dev)
        x, xf = _x(m, k, 2600 + m, dtype, dev)
        ref = oracle.gemm_quant(xf, blocks, qtype, n, k)
        bound = 4e-3 if dtype == "bfloat16" else 6e-4        # output rounding of bf16 (2^-9) / fp16 (2^-11)
        for variant in _configs():
            try:
                y = kernels.gemm_rcr(x, bq, qtype, variant=variant)
            except RuntimeError as exc:
                # a configuration may refuse a shape (the 8-bit-float ones keep K * M activation bytes in shared memory)
                assert "shape outside" in str(exc) and ":" in variant, (variant, m, n, k, str(exc))
                continue
            assert kernels.device_status() == 0, (variant, m, n, k)
            _, rel, norm = oracle.max_errors(ref, y.float().cpu().numpy())
            assert norm <= bound and rel <= (2e-2 if dtype == "bfloat16" else 1e-3), (qtype, dtype, variant, m, n, k, rel, norm)


def test_stream_gemv_repeated_launches_are_bit_identical():
    """Back-to-back launches (programmatic dependent launch lets them overlap on the GPU) give the same bits each time."""
    dev = torch.device("cuda:0")
    n, k = 11008, 4096
    bq = S.random_blocks_torch("Q4_K", n, k, 77, dev)
    x = torch.randn(1, k, device=dev).to(torch.bfloat16)
    for variant in _configs():
        outs = [torch.empty(1, n, device=dev, dtype=torch.bfloat16) for _ in range(6)]
        for o in outs:
            kernels.gemm_rcr(x, bq, "Q4_K", variant=variant, out=o)
        torch.cuda.synchronize()
        assert kernels.device_status() == 0
        for o in outs[1:]:
            assert torch.equal(o.view(torch.int16), outs[0].view(torch.int16)), variant
        want = kernels.gemm_rcr(x, bq, "Q4_K", variant="simt")
        assert float((outs[0].float() - want.float()).abs().max()) <= 2e-2 * float(want.float().abs().max())


@pytest.mark.parametrize("qtype", ["Q4_K", "Q6_K", "Q5_K", "Q4_0", "MXFP4", "NVFP4", "Q2_K", "Q3_K"])
def test_stream_gemv_bias_gated_and_scatter_epilogues(qtype):
    dev = torch.device("cuda:0")
    lib = _native.lib()
    k = 2048
    qv = {"Q4_K": 12, "Q6_K": 14, "Q5_K": 13, "Q4_0": 2, "MXFP4": 39, "NVFP4": 40, "Q2_K": 10, "Q3_K": 11}[qtype]
    for (m, n) in [(1, 104), (2, 64), (4, 200), (8, 48), (1, 3000)]:
        b0 = S.random_blocks(qtype, n, k, seed=2700 + n)
        b1 = S.random_blocks(qtype, n, k, seed=2800 + n)
        x, xf = _x(m, k, 2900 + m, "bfloat16", dev)
        # bias
        bias = torch.randn(n, device=dev, dtype=torch.bfloat16)
        ref = oracle.gemm_quant(xf, b0, qtype, n, k) + bias.float().cpu().numpy()
        y = kernels.gemm_rcr(x, torch.from_numpy(b0).to(dev), qtype, bias, variant="stream")
        _, _, norm = oracle.max_errors(ref, y.float().cpu().numpy())
        assert norm <= 4e-3, ("bias", m, n, norm)
        # gated dual GEMM on the row-interleaved pair
        w = kernels.interleave_rows8(torch.from_numpy(b0).to(dev), torch.from_numpy(b1).to(dev))
        for act in ("silu", "fast_gelu"):
            refg = oracle.dual_gemm_quant(xf, b0, b1, qtype, n, k, act)
            yg = kernels.dual_gemm_rcr(x, w, qtype, act, variant="stream")
            _, _, norm = oracle.max_errors(refg, yg.float().cpu().numpy())
            assert yg.shape == (m, n) and norm <= 2e-2, (act, m, n, norm)
        # scatter: the same values in every extra destination
        want = kernels.gemm_rcr(x, torch.from_numpy(b0).to(dev), qtype, variant="stream")
        dst = [torch.full((m, n), float("nan"), device=dev, dtype=torch.bfloat16) for _ in range(3)]
        peers = (ctypes.c_void_p * 2)(dst[1].data_ptr(), dst[2].data_ptr())
        rc = lib.dinoml_b200_gguf_gemm_rcr_scatter(x.data_ptr(), torch.from_numpy(b0).to(dev).data_ptr(), None, dst[0].data_ptr(), peers, 2, qv, 6,
                                                   m, n, k, _native.variant_code("stream"), torch.cuda.current_stream().cuda_stream)
        assert rc == 0, _native.last_error()
        torch.cuda.synchronize()
        for t in dst:
            assert torch.equal(t.view(torch.int16), want.view(torch.int16)), (m, n)
    assert kernels.device_status() == 0


def test_stream_variant_refusals():
    dev = torch.device("cuda:0")
    bq = torch.from_numpy(S.random_blocks("Q4_K", 32, 512, seed=3)).to(dev)
    with pytest.raises(RuntimeError, match="shape outside"):
        kernels.gemm_rcr(torch.zeros(9, 512, device=dev, dtype=torch.bfloat16), bq, "Q4_K", variant="stream")
    with pytest.raises(RuntimeError, match="shape outside"):
        kernels.gemm_rcr(torch.zeros(1, 512, device=dev, dtype=torch.bfloat16), bq, "Q4_K", variant="stream:99")
    with pytest.raises(RuntimeError, match="shape outside"):        # tuning configurations belong to the stream family only
        kernels.gemm_rcr(torch.zeros(1, 512, device=dev, dtype=torch.bfloat16), bq, "Q4_K", variant="mma:1")
    with pytest.raises(RuntimeError, match="unsupported dtype"):
        kernels.gemm_rcr(torch.zeros(1, 512, device=dev, dtype=torch.float32), bq, "Q4_K", variant="stream")
    assert not kernels.variant_supports("stream", "Q4_K", "bfloat16", 9, 32, 512)
    assert kernels.variant_supports("stream", "Q4_K", "bfloat16", 8, 32, 512)


@pytest.mark.parametrize("qtype", ["Q2_K", "Q3_K", "MXFP4"])
def test_stream_gemv_rows_that_are_not_16_byte_multiples_stay_with_simt(qtype):
    dev = torch.device("cuda:0")
    bad_k = {"Q2_K": 768, "Q3_K": 1024, "MXFP4": 768}[qtype]
    assert not kernels.variant_supports("stream", qtype, "bfloat16", 1, 64, bad_k)
    xk = torch.zeros(1, bad_k, device=dev, dtype=torch.bfloat16)
    with pytest.raises(RuntimeError):
        kernels.gemm_rcr(xk, S.random_blocks_torch(qtype, 64, bad_k, 1, dev), qtype, variant="stream")
    assert kernels.select_variant(qtype, "bfloat16", 1, 64, bad_k) == "simt"
